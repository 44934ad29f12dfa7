"""Mefupel configuration, from the keys of its config.json.

The file lists the layers one by one and may say that a run of them repeats with the same weights::

    {"architecture": "Mefupel", "vocab": V, "width": W, "norm": {"eps": e},
     "loop": {"start": a, "stop": b, "times": n} | null,
     "layers": [{"type": "attention",
                 "mixer": {"heads": H, "kv_heads": G, "dim": d, "vdim": dv, "scale": s, "mask": {"size": w} | null,
                           "rot": {"base": b, "dims": r}},
                 "mlp": {"kind": "dense", "ff": F} | null},
                {"type": "gla", "mixer": {"heads": H, "dim": d, "vdim": dv, "tau": t}, "mlp": ...},
                {"type": "parallel",
                 "mixer": {"left": {"heads": H, "kv_heads": G, "dim": d, "vdim": d, "scale": s, "mask": {"size": w} | null,
                                    "rot": {"base": b, "dims": r}},
                           "right": {"heads": H, "dim": d, "vdim": dv, "decay": [g_0, ...], "rot": {"base": b, "dims": r}}},
                 "mlp": ...}, ...]}

Every size and constant is read from there; a layer may differ from the next in all of them.  ``loop`` left out or null
is no repetition, ``mask`` left out or null an attention over all earlier tokens, ``mlp`` null a layer without a
feed-forward.  The rank of the low-rank projection behind a "gla" mixer's decay is not in the file: it is the shape of
the tensor (``rank``, optional, names it for a model that is written from a configuration).  ``max_positions``
(optional) bounds a sequence's length.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any

from .base import ConfigError, KeyReader, ModelConfig

MIXER_TYPES = ("attention", "gla", "parallel")
MLP_KINDS = ("dense",)
DEFAULT_MAX_POSITIONS = 1 << 20      # the design itself has no limit: positions are turned into angles on the fly


@dataclass(frozen=True)
class Rotation:
    base: float
    dims: int

    @classmethod
    def from_dict(cls, data, where):
        if not isinstance(data, dict):
            raise ConfigError(f"{where}: required key 'rot' is missing")
        r = KeyReader(data, where + ".rot")
        out = cls(base=r.number("base", positive=True), dims=r.integer("dims", minimum=0))
        if out.dims % 2:
            raise ConfigError(f"{where}.rot: 'dims' must be even (lanes turn in pairs)")
        return out

    def to_dict(self):
        return {"base": self.base, "dims": self.dims}


def _window(data, where) -> int:
    mask = data.get("mask")
    if mask is None:
        return 0
    return KeyReader(mask, where + ".mask").integer("size", minimum=1)


@dataclass(frozen=True)
class AttentionSpec:
    """Softmax attention over a sliding window: the "attention" mixer, and the left branch of a "parallel" one."""
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: int            # 0: every earlier token is seen
    rot: Rotation

    @classmethod
    def from_dict(cls, data, where):
        r = KeyReader(data, where)
        heads = r.integer("heads", minimum=1)
        out = cls(heads=heads, kv_heads=r.integer("kv_heads", heads, minimum=1), dim=r.integer("dim", minimum=1),
                  vdim=r.integer("vdim", minimum=1), scale=r.number("scale"), window=_window(data, where),
                  rot=Rotation.from_dict(data.get("rot"), where))
        if out.heads % out.kv_heads:
            raise ConfigError(f"{where}: 'kv_heads' must divide 'heads'")
        if out.rot.dims > out.dim:
            raise ConfigError(f"{where}.rot: {out.rot.dims} turning lanes in heads of {out.dim}")
        return out

    def to_dict(self):
        d = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim, "scale": self.scale,
             "rot": self.rot.to_dict()}
        if self.window:
            d["mask"] = {"size": self.window}
        return d


@dataclass(frozen=True)
class GlaSpec:
    heads: int
    dim: int
    vdim: int
    tau: float
    rank: int = 0          # of the decay's low-rank projection; 0: whatever the tensor's shape says

    @classmethod
    def from_dict(cls, data, where):
        r = KeyReader(data, where)
        return cls(heads=r.integer("heads", minimum=1), dim=r.integer("dim", minimum=1), vdim=r.integer("vdim", minimum=1),
                   tau=r.number("tau", positive=True), rank=r.integer("rank", 0, minimum=0) or 0)

    def to_dict(self):
        d = {"heads": self.heads, "dim": self.dim, "vdim": self.vdim, "tau": self.tau}
        if self.rank:
            d["rank"] = self.rank
        return d


@dataclass(frozen=True)
class RetentionSpec:
    heads: int
    dim: int
    vdim: int
    decay: tuple
    rot: Rotation

    @classmethod
    def from_dict(cls, data, where):
        r = KeyReader(data, where)
        decay = data.get("decay")
        if not isinstance(decay, list) or not all(isinstance(x, (int, float)) and not isinstance(x, bool) for x in decay):
            raise ConfigError(f"{where}: 'decay' must be a list of numbers, one per head")
        out = cls(heads=r.integer("heads", minimum=1), dim=r.integer("dim", minimum=1), vdim=r.integer("vdim", minimum=1),
                  decay=tuple(float(x) for x in decay), rot=Rotation.from_dict(data.get("rot"), where))
        if len(out.decay) != out.heads:
            raise ConfigError(f"{where}: {len(out.decay)} decays for {out.heads} heads")
        if out.rot.dims > out.dim:
            raise ConfigError(f"{where}.rot: {out.rot.dims} turning lanes in heads of {out.dim}")
        return out

    def to_dict(self):
        return {"heads": self.heads, "dim": self.dim, "vdim": self.vdim, "decay": list(self.decay), "rot": self.rot.to_dict()}


@dataclass(frozen=True)
class ParallelSpec:
    left: AttentionSpec
    right: RetentionSpec

    @classmethod
    def from_dict(cls, data, where):
        for key in ("left", "right"):
            if not isinstance(data.get(key), dict):
                raise ConfigError(f"{where}: required key '{key}' is missing")
        out = cls(AttentionSpec.from_dict(data["left"], where + ".left"), RetentionSpec.from_dict(data["right"], where + ".right"))
        if out.left.vdim != out.left.dim:
            raise ConfigError(f"{where}.left: the keys double as values, so 'vdim' must equal 'dim'")
        return out

    def to_dict(self):
        return {"left": self.left.to_dict(), "right": self.right.to_dict()}


MIXER_SPECS = {"attention": AttentionSpec, "gla": GlaSpec, "parallel": ParallelSpec}


@dataclass(frozen=True)
class MefupelMlp:
    kind: str
    ff: int

    @classmethod
    def from_dict(cls, data, where):
        r = KeyReader(data, where)
        kind = r.string("kind")
        if kind not in MLP_KINDS:
            raise ConfigError(f"{where}: kind '{kind}' is not one of {MLP_KINDS}")
        return cls(kind, ff=r.integer("ff", minimum=1))

    def to_dict(self):
        return {"kind": self.kind, "ff": self.ff}


@dataclass(frozen=True)
class MefupelLayer:
    type: str
    mixer: Any
    mlp: MefupelMlp | None = None

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
                   None if mlp is None else MefupelMlp.from_dict(mlp, where + ".mlp"))

    def to_dict(self):
        return {"type": self.type, "mixer": self.mixer.to_dict(), "mlp": None if self.mlp is None else self.mlp.to_dict()}


@dataclass(frozen=True)
class MefupelConfig(ModelConfig):
    vocab: int
    width: int
    layers: tuple
    norm_eps: float = 1e-5
    loop_start: int = 0
    loop_stop: int = 0
    loop_times: int = 1              # layers loop_start .. loop_stop - 1 run this many times in a row
    has_loop: bool = False           # whether the file names a loop at all (and the checkpoint a vector per pass)
    max_positions: int = DEFAULT_MAX_POSITIONS
    architecture: str = "Mefupel"
    extra: dict = field(default_factory=dict, compare=False)

    def __post_init__(self):
        object.__setattr__(self, "layers", tuple(self.layers))
        if not self.layers:
            raise ConfigError("a model needs at least one layer")
        if not (0 <= self.loop_start <= self.loop_stop <= len(self.layers)) or self.loop_times < 1:
            raise ConfigError(f"config.json.loop: layers {self.loop_start} .. {self.loop_stop} x {self.loop_times} "
                              f"of {len(self.layers)} layers")

    def runs(self) -> tuple:
        """(layer, number of the pass this run opens or None) in running order, the looped layers as often as they run."""
        n, a, b = len(self.layers), self.loop_start, self.loop_stop
        out = [(i, None) for i in range(a)]
        for t in range(self.loop_times if b > a else 0):
            out += [(i, t if i == a else None) for i in range(a, b)]
        return tuple(out + [(i, None) for i in range(b, n)])

    @classmethod
    def from_dict(cls, data: dict[str, Any]) -> "MefupelConfig":
        r = KeyReader(data)
        layers = data.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        norm = KeyReader(data.get("norm") or {}, "config.json.norm")
        loop = dict(loop_start=0, loop_stop=0, loop_times=1, has_loop=False)
        if data.get("loop") is not None:
            lr = KeyReader(data["loop"], "config.json.loop")
            loop = dict(loop_start=lr.integer("start", minimum=0), loop_stop=lr.integer("stop", minimum=0),
                        loop_times=lr.integer("times", 1, minimum=1), has_loop=True)
        return cls(vocab=r.integer("vocab", minimum=1), width=r.integer("width", minimum=1),
                   layers=tuple(MefupelLayer.from_dict(l, f"config.json.layers[{i}]") for i, l in enumerate(layers)),
                   norm_eps=norm.number("eps", positive=True),
                   max_positions=r.integer("max_positions", DEFAULT_MAX_POSITIONS, minimum=1),
                   architecture=r.string("architecture", "Mefupel"), **loop)

    def to_dict(self) -> dict[str, Any]:
        d = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.norm_eps},
             "layers": [l.to_dict() for l in self.layers]}
        if self.has_loop:
            d["loop"] = {"start": self.loop_start, "stop": self.loop_stop, "times": self.loop_times}
        if self.max_positions != DEFAULT_MAX_POSITIONS:
            d["max_positions"] = self.max_positions
        return d
